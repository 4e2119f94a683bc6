"""The Kolotar decoders on the hybrid engine (pipelinerl_b200/hybrid.py and its kernels) against
oracle/kolotar_oracle.py: each mechanism alone, whole prompts against token-by-token decoding, portions down to two
tokens, unequal batches against each request alone, pages and slots that are given back and taken again, the edges of
the sliding windows and of the query temperature's steps in prompts and in decoding, the sink, the blended values, far
tokens in the sums without a softmax and in the delta-rule memory, the first tokens, long decoding, awkward sizes, the
bf16 serving mode, greedy generation through the engine's scheduler, and the trace runner."""
import copy
import json
import subprocess
import sys

import pytest
import torch

from tests import kolotar_cases as kc

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4      # fp32 kernels against the float64 oracle
BF16_TOL = 8e-2     # bf16 operands / cache: rounding of activations dominates
A, T, P, M = kc.attention, kc.latent, kc.parallel, kc.moe


# ---- each mechanism alone ---------------------------------------------------------------------------------------
def _mechanisms():
    return {
        "attention": kc.model([A()]),
        "attention_every_head_its_own_keys_plain_rotation": kc.model([A(heads=4, kv_heads=4, dim=8, vdim=8, rot_dims=8, scaling=None, window=0)]),
        "attention_one_key_head_two_rotated_pairs": kc.model([A(heads=5, kv_heads=1, dim=14, vdim=6, rot_dims=4, window=7)]),
        "attention_window_of_one": kc.model([A(window=1)]),
        "attention_window_of_a_page": kc.model([A(window=64, scaling=(16.0, 32, 4.0, 0.5))]),
        "attention_values_blended_twice": kc.model([A(), A(v_mix=False), A(mlp=M()), A(window=3)]),
        "attention_wide_heads": kc.model([A(heads=2, kv_heads=1, dim=80, vdim=72, rot_dims=80, base=1e4)], width=40),
        "latent": kc.model([T()]),
        "latent_one_head_no_window": kc.model([T(heads=1, dim=5, rot_dim=14, vdim=9, kv_rank=11, base=7.0, window=0)]),
        "latent_two_rotated_channels": kc.model([T(heads=5, dim=16, rot_dim=2, vdim=8, kv_rank=40, window=3)]),
        "latent_wide_latent": kc.model([T(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=300, window=70)], width=48),
        "parallel": kc.model([P()]),
        "parallel_own_keys_no_temperature_no_cap": kc.model([P(heads=3, kv_heads=3, q_temp=None, softcap=0.0, r_heads=2, r_kv_heads=2)]),
        "parallel_shared_keys_one_tap": kc.model([P(heads=6, kv_heads=1, dim=7, vdim=5, r_heads=6, r_kv_heads=1, r_dim=9, r_vdim=33, conv=1)]),
        "parallel_temperature_every_token": kc.model([P(q_temp=(1.5, 1), heads=2, kv_heads=2, conv=2)]),
        "parallel_wide_delta_heads": kc.model([P(r_heads=2, r_kv_heads=1, r_dim=130, r_vdim=20, conv=5)], width=56),
        "parallel_many_heads": kc.model([P(heads=12, kv_heads=4, dim=6, vdim=4, r_heads=9, r_kv_heads=3, r_dim=4, r_vdim=5, conv=8)]),
        "routed_top2": kc.model([T(mlp=M())]),
        "routed_top1_of_seven": kc.model([A(mlp=M(experts=7, top=1, ff=10))]),
        "routed_all_experts": kc.model([P(mlp=M(experts=3, top=3, ff=9))]),
        "odd_width": kc.model([A(mlp=M()), P(mlp=M(experts=2, top=1, ff=7)), T()], vocab=61, width=50, alpha=0.5),
        "every_kind_in_another_order": kc.model([P(mlp=M()), T(), A(mlp=M()), P(heads=2, kv_heads=1), A(heads=3, kv_heads=3, vdim=10)],
                                                alpha=1.0),
    }


@pytest.mark.parametrize("name", sorted(_mechanisms()))
def test_each_mechanism_matches_the_oracle_fp32(cuda_device, name):
    config = _mechanisms()[name]
    wt = kc.weights(config, seed=len(name))
    toks = kc.tokens_for(config, 150)
    ref = kc.oracle_logits(config, wt, toks)
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    assert kc.rel_err(kc.stream_logits(eng, toks, [150]), ref) < F32_TOL
    assert kc.rel_err(kc.stream_logits(eng, toks, [2, 3, 61, 2, 7, 64, 2]), ref) < F32_TOL     # then one by one
    # the residual stream after every layer of a whole prompt
    res = kc.oracle_layers(config, wt, toks[:20])
    s = kc.stage_stream(eng, toks[:20])
    got = []
    eng._forward_rows([(s, 0, 20)], [], trace=got)
    eng.close_stream(s)
    assert len(got) == len(res)
    for a, b in zip(got, res):
        assert (a.double().cpu() - b).abs().max().item() < 1e-4 * max(1.0, b.abs().max().item())


FULL = kc.model([A(mlp=M()), P(mlp=M(experts=6, top=3, ff=16)), T(heads=2, dim=16, rot_dim=8, vdim=12, kv_rank=32, mlp=M()),
                 A(heads=3, kv_heads=3, dim=16, vdim=10, window=70), P(heads=2, kv_heads=1, r_heads=2, r_kv_heads=2, conv=4)],
                vocab=80, width=64)


def test_prefill_against_token_by_token_decoding(cuda_device):
    wt = kc.weights(FULL, 3)
    toks = kc.tokens_for(FULL, 140, seed=5)
    ref = kc.oracle_logits(FULL, wt, toks)
    eng = kc.build_engine(FULL, wt, torch.float32, cuda_device)
    whole = kc.stream_logits(eng, toks, [140])
    single = kc.stream_logits(eng, toks, [])                                 # every token alone, through the cache / state
    assert kc.rel_err(whole, ref) < F32_TOL and kc.rel_err(single, ref) < F32_TOL
    assert kc.rel_err(whole, single) < 2e-5


@pytest.mark.parametrize("portions", [[2] * 40, [63, 2, 63, 2], [64, 64], [1, 65, 1, 2, 59], [129, 2], [39, 1, 41, 9]])
def test_portions_of_several_sizes(cuda_device, portions):
    wt = kc.weights(FULL, 4)
    toks = kc.tokens_for(FULL, 140, seed=6)
    ref = kc.oracle_logits(FULL, wt, toks)
    eng = kc.build_engine(FULL, wt, torch.float32, cuda_device, prefill_chunk=96)   # 129 is cut by the engine too
    assert kc.rel_err(kc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_unequal_batches_equal_each_request_alone(cuda_device):
    wt = kc.weights(FULL, 7)
    seqs = [kc.tokens_for(FULL, n, seed=10 + n) for n in (1, 37, 130, 66)]
    eng = kc.build_engine(FULL, wt, torch.float32, cuda_device)
    alone = [kc.stream_logits(eng, s, [len(s)]) for s in seqs]
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
        assert kc.rel_err(torch.cat(got[i]), alone[i]) < 2e-5, f"request {i} depends on its batch"
    assert kc.rel_err(alone[2], kc.oracle_logits(FULL, wt, seqs[2])) < F32_TOL


def test_pages_and_slots_are_reused(cuda_device):
    """Two slots and five pages for eight sequences: every later sequence runs in a slot whose delta-rule memory and
    convolution inputs another one left, and on pages that held other keys, values and latents."""
    wt = kc.weights(FULL, 8)
    eng = kc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=192, n_pages=1 + 5)
    lens = [100, 70, 5, 128, 64, 1, 150, 65]
    for k, n in enumerate(lens):
        toks = kc.tokens_for(FULL, n, seed=40 + k)
        ref = kc.oracle_logits(FULL, wt, toks)
        held = eng.open_stream()
        eng.feed([(held, kc.tokens_for(FULL, 60 + k, seed=k), [])])          # a neighbour that dirties the other slot
        got = kc.stream_logits(eng, toks, [max(1, n // 2), 2])
        eng.close_stream(held)
        assert kc.rel_err(got, ref) < F32_TOL, f"sequence {k}"
        assert len(eng.free_pages) == 5 and len(eng.free_slots) == 2


# ---- edges made to stand out ------------------------------------------------------------------------------------------
def _with(config, path, value):
    """A copy of the config with one nested key replaced."""
    out = copy.deepcopy(config)
    node = out
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    return out


PLANS = ([330], [63, 1, 1, 63, 2, 126], [64, 64, 64, 64], [199, 2, 54, 2], [250])       # the rest one by one


@pytest.mark.parametrize("window", [33, 64, 65, 200])
def test_window_edges_of_softmax_attention(cuda_device, window):
    """Peaked scores (a large score scale) so that single keys carry a row's weight; the oracle with a window one longer
    or one shorter, and without the sink, is far outside the tolerance, so a key that is one position off at the edge
    shows, in portions of a prompt and in single decoded tokens, at page borders and inside pages."""
    config = kc.model([A(heads=4, kv_heads=2, dim=12, vdim=10, window=window, scale=1.2)], width=40)
    wt = kc.weights(config, 19)
    wt["l0.mix.sink"] = kc.bf16_round(wt["l0.mix.sink"] + 3.0)
    toks = kc.tokens_for(config, 330, seed=3)
    ref = kc.oracle_logits(config, wt, toks)
    for other in (window - 1, window + 1):
        wrong = kc.oracle_logits(_with(config, ["layers", 0, "mixer", "mask", "size"], other), wt, toks)
        assert kc.rel_err(wrong[window:], ref[window:]) > 100 * F32_TOL
        assert ((wrong - ref).abs().amax(-1)[window:] > 1e-4).float().mean() > 0.5        # most positions, not one
    no_sink = dict(wt)
    no_sink["l0.mix.sink"] = torch.full((4,), -1e4, dtype=torch.float64)
    assert kc.rel_err(kc.oracle_logits(config, no_sink, toks), ref) > 100 * F32_TOL
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in PLANS:
        assert kc.rel_err(kc.stream_logits(eng, toks, portions), ref) < F32_TOL
    eng16 = kc.build_engine(config, wt, torch.bfloat16, cuda_device)
    assert kc.rel_err(kc.stream_logits(eng16, toks, [199, 2, 54, 2]), ref) < BF16_TOL


@pytest.mark.parametrize("window", [2, 64, 129])
def test_window_edges_of_latent_attention(cuda_device, window):
    config = kc.model([T(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, window=window, scale=1.5)], width=40)
    wt = kc.weights(config, 21)
    toks = kc.tokens_for(config, 330, seed=4)
    ref = kc.oracle_logits(config, wt, toks)
    for other in (window - 1, window + 1):
        wrong = kc.oracle_logits(_with(config, ["layers", 0, "mixer", "mask", "size"], other), wt, toks)
        assert kc.rel_err(wrong[window:], ref[window:]) > 100 * F32_TOL
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in PLANS:
        assert kc.rel_err(kc.stream_logits(eng, toks, portions), ref) < F32_TOL
    eng16 = kc.build_engine(config, wt, torch.bfloat16, cuda_device)
    assert kc.rel_err(kc.stream_logits(eng16, toks, [199, 2, 54, 2]), ref) < BF16_TOL


def test_rotation_follows_the_position(cuda_device):
    """Fast rotations on every channel: a key or query turned by a neighbouring position's angle, pairs taken in the
    wrong layout, or a scaling that is left out move the scores by O(1)."""
    config = kc.model([A(heads=2, kv_heads=1, dim=12, vdim=10, rot_dims=12, base=3.0, scaling=(4.0, 16, 2.0, 0.25), window=90),
                       T(heads=2, dim=2, rot_dim=12, vdim=10, kv_rank=12, base=3.0, scale=1.5, window=0)], width=40)
    wt = kc.weights(config, 23)
    toks = kc.tokens_for(config, 200, seed=2)
    ref = kc.oracle_logits(config, wt, toks)
    for path, value in ((["layers", 0, "mixer", "rot", "base"], 3.3), (["layers", 1, "mixer", "rot", "base"], 3.3),
                        (["layers", 0, "mixer", "rot", "scaling", "factor"], 3.0), (["layers", 0, "mixer", "rot", "scaling", "fast"], 1.0)):
        assert kc.rel_err(kc.oracle_logits(_with(config, path, value), wt, toks), ref) > 100 * F32_TOL
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in ([200], [1, 2, 62, 3, 64], [130]):
        assert kc.rel_err(kc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_blended_values_come_from_the_first_such_layer(cuda_device):
    config = kc.model([A(v_mix=False), A(), A(v_mix=False), A(), A()], width=48)
    wt = kc.weights(config, 29)
    toks = kc.tokens_for(config, 100, seed=7)
    ref = kc.oracle_logits(config, wt, toks)
    for name in ("l3.mix.vmix", "l4.mix.vmix"):                               # each blend matters; the first layer's weight does not
        other = dict(wt)
        other[name] = torch.zeros((), dtype=torch.float64)
        assert kc.rel_err(kc.oracle_logits(config, other, toks), ref) > 100 * F32_TOL
    other = dict(wt)
    other["l1.mix.vmix"] = torch.zeros((), dtype=torch.float64)
    assert kc.rel_err(kc.oracle_logits(config, other, toks), ref) == 0.0
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in ([100], [30, 2, 5], []):
        assert kc.rel_err(kc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_far_tokens_without_a_softmax_and_the_temperature_steps(cuda_device):
    """Weights that are not normalised: every key of the past adds to the sum, so the first token still matters after
    300 more (a key that is lost or counted twice at a page border or at the start of a portion shows everywhere
    behind it).  The query temperature steps at positions every * k - 1; portions start and end on those positions."""
    config = kc.model([P(heads=4, kv_heads=2, q_temp=(2.0, 32), softcap=5.0, scale=0.8)], width=40)
    wt = kc.weights(config, 31)
    wt["l0.mix.left.pb"] = kc.bf16_round(wt["l0.mix.left.pb"] - 3.0)         # small weights: the sums stay O(1)
    toks = kc.tokens_for(config, 330, seed=9)
    ref = kc.oracle_logits(config, wt, toks)
    other = [(toks[0] + 1) % config["vocab"]] + toks[1:]
    assert kc.rel_err(kc.oracle_logits(config, wt, other)[300:], ref[300:]) > 20 * F32_TOL      # token 0 still matters
    for path, value in ((["layers", 0, "mixer", "left", "q_temp", "every"], 33), (["layers", 0, "mixer", "left", "q_temp", "coef"], 1.5),
                        (["layers", 0, "mixer", "left", "softcap"], 4.0)):
        assert kc.rel_err(kc.oracle_logits(_with(config, path, value), wt, toks), ref) > 100 * F32_TOL
    no_talk = dict(wt)
    no_talk["l0.mix.left.talk"] = torch.eye(4, dtype=torch.float64)
    assert kc.rel_err(kc.oracle_logits(config, no_talk, toks), ref) > 100 * F32_TOL
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in PLANS + ([31, 1, 31, 2, 63, 32],):
        assert kc.rel_err(kc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_far_tokens_in_the_delta_rule_memory(cuda_device):
    """Decays close to 1: the memory at token 300 still holds the first tokens, so a state (or the convolution's last
    inputs) that is lost, reset or not carried across portions shows at every later position.  A second model with
    strong decay exercises the other end."""
    config = kc.model([P(left_scale=0.05, right_scale=1.0, r_heads=4, r_kv_heads=2, r_dim=12, r_vdim=8, conv=4)], width=40)
    for shift, far in ((-6.0, True), (2.0, False)):
        wt = kc.weights(config, 11)
        wt["l0.mix.right.A_log"] = kc.bf16_round(wt["l0.mix.right.A_log"] + shift)
        toks = kc.tokens_for(config, 300, seed=4)
        ref = kc.oracle_logits(config, wt, toks)
        if far:
            other = [(toks[0] + 1) % config["vocab"]] + toks[1:]
            assert kc.rel_err(kc.oracle_logits(config, wt, other)[250:], ref[250:]) > 20 * F32_TOL
        eng = kc.build_engine(config, wt, torch.float32, cuda_device)
        assert kc.rel_err(kc.stream_logits(eng, toks, [300]), ref) < F32_TOL
        assert kc.rel_err(kc.stream_logits(eng, toks, [7, 2, 120, 2, 9]), ref) < F32_TOL      # then 160 single tokens
        assert kc.rel_err(kc.stream_logits(eng, toks, [1, 1, 1, 2, 3, 100]), ref) < F32_TOL   # portions shorter than the taps


def test_first_tokens_and_one_token_sequences(cuda_device):
    wt = kc.weights(FULL, 12)
    eng = kc.build_engine(FULL, wt, torch.float32, cuda_device)
    for n in (1, 2, 3, 4, 5):
        toks = kc.tokens_for(FULL, n, seed=70 + n)
        ref = kc.oracle_logits(FULL, wt, toks)
        assert kc.rel_err(kc.stream_logits(eng, toks, [n]), ref) < F32_TOL
        assert kc.rel_err(kc.stream_logits(eng, toks, []), ref) < F32_TOL


def test_routing_follows_the_logits_and_their_bias(cuda_device):
    """Eleven experts of which three are taken, router rows scaled so that the choice is never a close call and a bias
    large enough to change it: a wrong expert, weights normalised over all experts or a forgotten bias shows at once."""
    config = kc.model([T(mlp=M(experts=11, top=3, ff=12))], width=40)
    wt = kc.weights(config, 17)
    wt["l0.mlp.router"] = kc.bf16_round(wt["l0.mlp.router"] * 3.0)
    wt["l0.mlp.router.b"] = kc.bf16_round(wt["l0.mlp.router.b"] * 20.0)
    toks = kc.tokens_for(config, 120, seed=4)
    ref = kc.oracle_logits(config, wt, toks)
    other = dict(wt)
    other["l0.mlp.router.b"] = torch.zeros(11, dtype=torch.float64)
    assert kc.rel_err(kc.oracle_logits(config, other, toks), ref) > 50 * F32_TOL
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    assert kc.rel_err(kc.stream_logits(eng, toks, [100, 2]), ref) < F32_TOL
    eng.unfused_router = True
    assert kc.rel_err(kc.stream_logits(eng, toks, [100, 2]), ref) < F32_TOL


BIG = kc.model([A(heads=8, kv_heads=2, dim=32, vdim=32, rot_dims=16, window=100, mlp=M(experts=3, top=3, ff=64)),
                T(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=64, window=120, mlp=M(experts=3, top=3, ff=64)),
                P(heads=4, kv_heads=2, dim=32, vdim=32, r_heads=4, r_kv_heads=2, r_dim=64, r_vdim=32, conv=4,
                  mlp=M(experts=4, top=2, ff=96))], vocab=200, width=128)


@pytest.mark.parametrize("plain_gemm", [False, True])
def test_bf16_serving_mode(cuda_device, plain_gemm):
    """bf16 operands and cache with the tensor-core GEMMs (and with the CUDA-core GEMM) against the float64 oracle.  Only
    the last layer's router has a choice to make (the earlier ones take all their experts), so a token whose last-taken
    and first-left-out router logits are closer than bf16 rounding can tell apart touches only its own logits; the oracle
    reports the gaps and those positions are left out."""
    wt = kc.weights(BIG, 13)
    toks = kc.tokens_for(BIG, 300, seed=8)
    gaps = []
    ref = kc.oracle_logits(BIG, wt, toks, margins=gaps)
    assert len(gaps) == 3 and min(gaps[0].min().item(), gaps[1].min().item()) == float("inf")
    clear = gaps[-1] > 0.1
    assert clear.float().mean().item() > 0.8
    eng = kc.build_engine(BIG, wt, torch.bfloat16, cuda_device, prefill_chunk=512)
    eng.force_plain_gemm = plain_gemm
    whole = kc.stream_logits(eng, toks, [300])
    assert kc.rel_err(whole[clear], ref[clear]) < BF16_TOL
    assert kc.rel_err(kc.stream_logits(eng, toks, [100, 2, 30])[clear], ref[clear]) < BF16_TOL
    # the bf16 engine is about as close to the oracle as the oracle with only its matrix products' inputs rounded
    least = kc.rel_err(kc.oracle_logits(BIG, wt, toks, round_inputs=True)[clear], ref[clear])
    assert kc.rel_err(whole[clear], ref[clear]) < 3 * least + 1e-3


def test_long_decoding(cuda_device):
    """A short prompt and 400 single tokens over six page borders, in fp32 against the oracle."""
    config = kc.model([A(mlp=M(), window=150), P(), T(window=130)])
    wt = kc.weights(config, 31)
    toks = kc.tokens_for(config, 420, seed=12)
    eng = kc.build_engine(config, wt, torch.float32, cuda_device)
    assert kc.rel_err(kc.stream_logits(eng, toks, [20]), kc.oracle_logits(config, wt, toks)) < F32_TOL


def test_greedy_generation_through_the_scheduler(cuda_device):
    """add_request / run_prefill / CUDA-graph token steps / harvest, five prompts on two slots (slots and pages are
    reused, idle slots ride along in the step), greedy ids against the oracle wherever its top-2 margin is not a
    rounding matter."""
    from pipelinerl_b200.engine import SamplingParams
    wt = kc.weights(FULL, 14)
    eng = kc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=256, use_cuda_graph=True,
                          prefill_chunk=64)
    prompts = [kc.tokens_for(FULL, n, seed=90 + n) for n in (1, 5, 70, 130, 64)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, greedy=True, ignore_eos=True))
    assert len(eng.free_slots) == 2 and len(eng.free_pages) == eng.n_pages - 1
    for p, r in zip(prompts, outs):
        assert len(r.output_ids) == 6 and r.finish_reason == "length"
        seq = list(p)
        for tok, lp in zip(r.output_ids, r.output_logprobs):
            lg = kc.oracle_logits(FULL, wt, seq)[-1]
            top = torch.topk(lg, 2)
            if (top.values[0] - top.values[1]).item() > 1e-3:
                assert tok == top.indices[0].item()
            assert abs(lp - torch.log_softmax(lg, -1)[tok].item()) < 1e-3
            seq.append(tok)


def test_trace_runner_command_line(cuda_device, tmp_path):
    """bin/trace_run on a checkpoint folder: registry, safetensors loader, streams, output files, in both dtypes."""
    config = kc.model([A(mlp=M(experts=4, top=1, ff=8)), P(mlp=M(experts=3, top=2, ff=24)), T()], vocab=64, width=40)
    wt = kc.weights(config, 15)
    kc.write_checkpoint(tmp_path, config, wt)
    a, b = kc.tokens_for(config, 90, seed=1), kc.tokens_for(config, 20, seed=2)
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=a[:50], want=[0, 49])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=a[50:52], want=[]), dict(id="b", tokens=b[:19], want=[3])], end=[]),
        dict(step=2, entries=[dict(id="b", tokens=b[19:], want=[0]), dict(id="a", tokens=a[52:], want=[37])], end=["a", "b"]),
        dict(step=3, entries=[dict(id="c", tokens=b, want=[19])], end=["c"]),
    ]
    ra, rb = kc.oracle_logits(config, wt, a), kc.oracle_logits(config, wt, b)
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
            assert got.shape == ref.shape and kc.rel_err(got, ref) < tol


@pytest.mark.parametrize("dim,vdim,window", [(32, 32, 100), (64, 64, 64), (128, 128, 37), (80, 48, 90), (48, 96, 33), (16, 16, 200),
                                             (240, 128, 70)])
def test_tensor_core_prompt_attention_with_sink_and_window(cuda_device, dim, vdim, window):
    """bf16 with head sizes the tensor-core prompt kernel is built for (square ones and key sizes that differ from the
    value size): the sink joins its denominator after the last key tile.  Strong sinks and peaked scores over five page borders, against the CUDA-core kernel on the same cache (they
    differ by the bf16 rounding of the softmax weights) and against the oracle; then the latent layer's tensor-core
    kernel with its window, portions and single tokens."""
    config = kc.model([A(heads=4, kv_heads=2, dim=dim, vdim=vdim, rot_dims=dim // 2, window=window, scale=2.0 * dim ** -0.5),
                       T(heads=6, dim=16, rot_dim=16, vdim=24, kv_rank=32, window=window, scale=0.6)], width=64)
    wt = kc.weights(config, 9)
    wt["l0.mix.sink"] = kc.bf16_round(wt["l0.mix.sink"] * 2.0 + 3.0)
    toks = kc.tokens_for(config, 330, seed=3)
    ref = kc.oracle_logits(config, wt, toks)
    eng = kc.build_engine(config, wt, torch.bfloat16, cuda_device, prefill_chunk=512)
    assert eng.lib.prl_attn_latent_fits(48, 32, 64)
    plans = ([330], [63, 17, 16, 130, 65, 20, 3, 2], [300])                 # the rest one by one
    fast = [kc.stream_logits(eng, toks, p) for p in plans]
    eng.force_plain_attn = True
    eng.lib.prl_attn_any_tensor_cores(0)
    try:
        plain = [kc.stream_logits(eng, toks, p) for p in plans]
    finally:
        eng.lib.prl_attn_any_tensor_cores(1)
    for f, p in zip(fast, plain):
        assert 0 < kc.rel_err(f, p) < 0.25 * BF16_TOL                        # two kernels, the same result
        assert kc.rel_err(f, ref) < BF16_TOL and kc.rel_err(p, ref) < BF16_TOL


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 32, 32), (6, 3, 16, 64), (20, 4, 16, 128), (3, 1, 48, 128), (6, 2, 80, 48),
                                                      (2, 2, 16, 16), (5, 5, 32, 112), (32, 8, 128, 128)])
def test_tensor_core_attention_without_a_softmax(cuda_device, heads, kv_heads, dim, vdim):
    """bf16 with sizes the tensor-core kernel is built for (more output heads than one CTA holds in two cases, of which the
    last has queries too large to be staged beside the tiles): prompt
    portions, mixed batches and single tokens (whose keys are split over CTAs and added afterwards) against the
    CUDA-core kernel on the same cache (they differ by the bf16 rounding of the mixed weights) and against the oracle.
    Weights kept small by the head bias so that 330 unnormalised terms stay O(1)."""
    config = kc.model([P(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, q_temp=(0.7, 48), softcap=8.0, left_scale=1.0,
                         right_scale=0.1)], width=64)
    wt = kc.weights(config, 9)
    wt["l0.mix.left.pb"] = kc.bf16_round(wt["l0.mix.left.pb"] - 3.0)
    toks = kc.tokens_for(config, 330, seed=3)
    ref = kc.oracle_logits(config, wt, toks)
    eng = kc.build_engine(config, wt, torch.bfloat16, cuda_device, prefill_chunk=512)
    assert eng.lib.prl_attn_sigmoid_tc_fits(heads, kv_heads, dim, vdim)
    plans = ([330], [63, 17, 16, 130, 65, 20, 3, 2], [300])                 # the rest one by one
    fast = [kc.stream_logits(eng, toks, p) for p in plans]
    eng.force_plain_attn = True
    plain = [kc.stream_logits(eng, toks, p) for p in plans]
    for f, p in zip(fast, plain):
        assert 0 < kc.rel_err(f, p) < 0.25 * BF16_TOL
        assert kc.rel_err(f, ref) < BF16_TOL and kc.rel_err(p, ref) < BF16_TOL
    # a mixed batch: a portion beside single tokens of other sequences
    eng.force_plain_attn = False
    a, b, c = eng.open_stream(), eng.open_stream(), eng.open_stream()
    eng.feed([(b, toks[:70], []), (c, toks[:129], [])])
    got = eng.feed([(a, toks[:100], list(range(100))), (b, toks[70:71], [0]), (c, toks[129:130], [0])]).double().cpu()
    assert kc.rel_err(got[:100], ref[:100]) < BF16_TOL and kc.rel_err(got[100:101], ref[70:71]) < BF16_TOL
    assert kc.rel_err(got[101:], ref[129:130]) < BF16_TOL
    for s in (a, b, c):
        eng.close_stream(s)
