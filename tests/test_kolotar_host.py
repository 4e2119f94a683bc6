"""Host-side checks of the Kolotar family (no GPU): the config parser, the fused arena layout against the checkpoint
names, the registry, the rotary table, and the oracle's own consistency."""
import math

import pytest
import torch

from oracle import kolotar_oracle as ko
from tests import kolotar_cases as kc


def _config():
    return kc.model([kc.parallel(mlp=kc.moe()), kc.attention(mlp=kc.moe(experts=4, top=1, ff=8)), kc.latent(heads=2, dim=8, rot_dim=4),
                     kc.attention(v_mix=False, window=0), kc.attention(heads=3, kv_heads=3, dim=16, vdim=10)])


def test_the_parser_reads_every_constant():
    from pipelinerl_b200.hybrid import HybridConfig
    config = _config()
    cfg = HybridConfig.from_kolotar(config, ko.tensor_shapes(config))
    assert [L.kind for L in cfg.layers] == ["sigmoid_delta", "attention", "latent_attention", "attention", "attention"]
    assert cfg.block == "post_ln" and cfg.skip_scale == 2.5 and cfg.tied_head and "head" not in dict(cfg.fused_shapes())
    left, right = cfg.layers[0].attn, cfg.layers[0].gdelta
    assert (left.weights, left.q_temp, left.softcap, left.talking, left.heads, left.kv_heads) == ("sigmoid", (0.5, 16.0), 20.0, True, 4, 2)
    assert (right.heads, right.kv_heads, right.dim, right.vdim, right.conv) == (4, 2, 12, 8, 3)
    assert (cfg.layers[0].left_scale, cfg.layers[0].right_scale) == (0.7, 0.6)
    a = cfg.layers[1].attn
    assert (a.window, a.rot_dims, a.rot_half, a.rot_scaling, a.sink, a.v_norm, a.gate_per_head) == (40, 8, True, (3.0, 64.0, 8.0, 1.0), True, True, True)
    assert [L.attn.v_mix for L in cfg.layers if L.kind == "attention"] == [1, 0, 2]      # keeps, none, blends
    t = cfg.layers[2].latent
    assert (t.q_rank, t.interleaved, t.window, t.sink, t.gate) == (0, True, 50, False, True)
    moe = cfg.layers[1].mlp.moe
    assert (moe.score, moe.weight_on, moe.router_bias, moe.top, moe.experts) == ("softmax_top", "output", True, 1, 4)
    assert cfg.layers[2].mlp is None


def test_every_checkpoint_tensor_has_a_place_in_the_arena():
    from pipelinerl_b200.hybrid import HybridConfig
    config = _config()
    shapes = ko.tensor_shapes(config)
    cfg = HybridConfig.from_kolotar(config, shapes)
    slices, fused = cfg.checkpoint_slices(), dict(cfg.fused_shapes())
    assert set(slices) == set(shapes)
    covered = {}
    for name, (dst, r0, rn) in slices.items():
        shape = shapes[name] or (1,)
        assert (rn, *shape[1:]) == (shape[0], *fused[dst][1:]), name
        covered.setdefault(dst, []).append((r0, rn))
    for dst, spans in covered.items():                      # the slices tile every fused tensor exactly
        at = 0
        for r0, rn in sorted(spans):
            assert r0 == at
            at += rn
        assert at == fused[dst][0], dst
    assert set(covered) == set(fused)
    # without a file every optional tensor is assumed (a blending weight only where it is used); a checkpoint without
    # the optional ones parses too
    assert dict(HybridConfig.from_kolotar(config).fused_shapes()).keys() == fused.keys() - {"l1.mix.vmix", "l3.mix.vmix"}
    bare = {k: v for k, v in shapes.items() if not k.endswith((".sink", "router.b", "mix.o.b")) and k != "l1.mix.vmix"}
    cfg2 = HybridConfig.from_kolotar(config, bare)
    assert set(cfg2.checkpoint_slices()) == set(bare) and not cfg2.layers[1].attn.sink and not cfg2.layers[1].mlp.moe.router_bias


def test_bad_sizes_are_refused():
    from pipelinerl_b200.hybrid import HybridConfig
    for bad in (kc.model([kc.attention(heads=5, kv_heads=2)]), kc.model([kc.attention(rot_dims=7)]), kc.model([kc.attention(rot_dims=14)]),
                kc.model([kc.latent(rot_dim=5)]), kc.model([kc.parallel(r_heads=3, r_kv_heads=2)]), kc.model([kc.parallel(conv=0)]),
                kc.model([kc.attention(), kc.attention(kv_heads=2)]),                       # blended values of another size
                kc.model([kc.latent(mlp=kc.moe(experts=2, top=3))])):
        with pytest.raises(ValueError):
            HybridConfig.from_kolotar(bad)
    odd = kc.model([kc.attention()])
    odd["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError):
        HybridConfig.from_kolotar(odd)


def test_registry_knows_the_architecture(tmp_path):
    from pipelinerl_b200 import registry
    config = _config()
    kc.write_checkpoint(tmp_path, config, kc.weights(config, 1))
    fam, cfg = registry.load_config(tmp_path)
    assert fam.name == "Kolotar" and torch.float32 in fam.dtypes and torch.bfloat16 in fam.dtypes
    assert cfg.vocab_size == config["vocab"] and len(cfg.layers) == 5


def test_rotary_table_matches_the_oracle_and_its_limits():
    from pipelinerl_b200.hybrid import rotary_table
    for dims, base, sc in ((8, 50.0, (3.0, 64, 8.0, 1.0)), (64, 1e6, (8.0, 1024, 16.0, 2.0)), (12, 3.0, (4.0, 16, 2.0, 0.25)),
                           (16, 1e4, None), (2, 10.0, (2.0, 8, 4.0, 1.0))):
        f, mag = rotary_table(dims, base, sc)
        ref, rmag = ko.rotary_frequencies(dims, base, dict(factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3]) if sc else None)
        assert torch.allclose(torch.tensor(f, dtype=torch.float64), ref, rtol=1e-14, atol=0) and mag == rmag
        plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        if sc:          # every pair lies between its plain frequency and that divided by the factor
            assert all(p / sc[0] * (1 - 1e-12) <= x <= p * (1 + 1e-12) for x, p in zip(f, plain))
            assert mag == 0.1 * math.log(sc[0]) + 1.0
        else:
            assert f == plain and mag == 1.0
    assert rotary_table(0, 10.0, None) == ([], 1.0)


def test_oracle_mechanisms_agree_with_their_definitions():
    g = torch.Generator().manual_seed(0)
    T, H, G, d, dv = 9, 4, 2, 6, 5
    q, k, v = (torch.randn(T, n, e, generator=g, dtype=torch.float64) for n, e in ((H, d), (G, d), (G, dv)))
    # a window of one sees only the token itself: the output is its own value, scaled by the sink's share
    sink = torch.tensor([0.3, -1.0, 2.0, 0.0], dtype=torch.float64)
    o = ko.softmax_attention(q, k, v, 0.4, 1, sink)
    for h in range(H):
        s = (q[:, h] * k[:, h // 2]).sum(-1) * 0.4
        share = torch.exp(s) / (torch.exp(s) + torch.exp(sink[h]))
        assert torch.allclose(o[:, h], share[:, None] * v[:, h // 2], atol=1e-12)
    # without a softmax, an identity mixing matrix and zero scores every visible key weighs sigmoid(b): a running sum
    o = ko.sigmoid_attention(torch.zeros_like(q), k, v, 1.0, 0.0, torch.zeros(H, dtype=torch.float64), torch.eye(H, dtype=torch.float64))
    assert torch.allclose(o[:, 1], 0.5 * torch.cumsum(v[:, 0], 0), atol=1e-12)
    # the gated delta rule with beta = 1, g = 1 and orthonormal keys stores each value under its key
    keys = torch.eye(4, dtype=torch.float64)[:, None, :]
    vals = torch.randn(4, 1, 3, generator=g, dtype=torch.float64)
    ones = torch.ones(4, 1, dtype=torch.float64)
    o = ko.gated_delta_rule(keys, keys, vals, ones, ones)
    assert torch.allclose(o, vals, atol=1e-12)                                        # read back with its own key at once
    o = ko.gated_delta_rule(keys[[0, 1, 2, 0]], keys[[0, 1, 2, 0]], vals, ones, ones)
    assert torch.allclose(o[3], vals[3], atol=1e-12)                                  # writing key 0 again replaces its value
    # the convolution's last tap is the current token's
    x = torch.randn(5, 2, generator=g, dtype=torch.float64)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = ko.causal_conv_silu(x, taps)
    assert torch.allclose(y[:, 0], x[:, 0] * torch.sigmoid(x[:, 0])) and torch.allclose(y[:2, 1], torch.zeros(2, dtype=torch.float64))
    assert torch.allclose(y[2:, 1], x[:3, 1] * torch.sigmoid(x[:3, 1]))
    # both rotations keep lengths (up to the scaling's factor) and make scores depend on the distance only
    f, mag = ko.rotary_frequencies(6, 20.0, dict(factor=2.0, original=8, fast=2.0, slow=0.5))
    a, b = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    for rot in (lambda x, p: ko.rotate_half(x, torch.tensor([p]), f, mag, 6), lambda x, p: ko.rotate_pairs(x, torch.tensor([p]), f, 6) * mag):
        assert torch.allclose((rot(a, 5) * rot(b, 3)).sum(), (rot(a, 12) * rot(b, 10)).sum(), atol=1e-12)
        assert torch.allclose(rot(a, 7)[..., 6:], a[..., 6:] * (1.0 if rot(a, 0)[..., 7] == a[..., 7] else mag))
        assert torch.allclose(rot(a, 7)[..., :6].norm(), a[..., :6].norm() * mag, atol=1e-12)
