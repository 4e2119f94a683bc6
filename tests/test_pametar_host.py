"""Host-side checks of the Pametar family (no GPU): the config parser, the fused arena layout against the checkpoint
names, the registry, and the oracle's own consistency."""
import json

import pytest
import torch

from oracle import pametar_oracle as po
from tests import pametar_cases as pc


def _config():
    return pc.model([pc.latent(mlp=pc.moe()), pc.delta(mlp=pc.moe(experts=4, top=1, ff=8)), pc.latent(heads=2, dim=8, rot_dim=4)],
                    loop=(0, 2, 3), streams=3)


def test_layer_runs_unroll_the_repeated_block():
    from pipelinerl_b200.hybrid import HybridConfig
    cfg = HybridConfig.from_pametar(_config())
    assert [L.weights_of for L in cfg.layers] == [0, 1, 0, 1, 0, 1, 2] == po.layer_runs(_config())
    assert [L.kind for L in cfg.layers][:2] == ["latent", "delta"] and cfg.streams == 3 and cfg.norm_kind == "tanh"
    assert cfg.pair_embed == (53, 11, 5)
    moe = cfg.layers[0].mlp.moe
    assert (moe.score, moe.weight_on, moe.weight_scale, moe.top) == ("softmax_all", "output", 1.5, 2)
    assert cfg.layers[1].delta.rank == 5 and abs(cfg.layers[1].delta.decay_scale - 0.6065306597) < 1e-9


@pytest.mark.parametrize("parts", [{}, dict(layer_scale=False), dict(gated=False), dict(sink=False)])
def test_every_checkpoint_tensor_has_a_place_in_the_arena(parts):
    from pipelinerl_b200.hybrid import HybridConfig
    config = _config()
    shapes = po.tensor_shapes(config, **parts)
    cfg = HybridConfig.from_pametar(config, shapes)
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


def test_streams_need_their_weights_and_sizes_are_checked():
    from pipelinerl_b200.hybrid import HybridConfig
    config = _config()
    with pytest.raises(ValueError):
        HybridConfig.from_pametar(config, po.tensor_shapes(config, hyper=False))       # three streams, no stream weights
    one = pc.model([pc.delta()], streams=1)
    assert not HybridConfig.from_pametar(one, po.tensor_shapes(one, hyper=False)).layers[0].hyper
    bad = pc.model([pc.latent(rot_dim=5)])
    with pytest.raises(ValueError):
        HybridConfig.from_pametar(bad)
    bad = pc.model([pc.latent(kv_rank=600)])
    with pytest.raises(ValueError):
        HybridConfig.from_pametar(bad)
    bad = _config()
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        HybridConfig.from_pametar(bad)


def test_registry_reads_a_checkpoint_folder(tmp_path):
    from pipelinerl_b200 import registry
    config = _config()
    wt = pc.weights(config, 2)
    pc.write_checkpoint(tmp_path, config, wt)
    fam, cfg = registry.load_config(tmp_path)
    assert fam.name == "Pametar" and torch.float32 in fam.dtypes and torch.bfloat16 in fam.dtypes
    assert cfg.num_params() == sum(max(1, v.numel()) for v in wt.values())
    back = registry.read_safetensors(tmp_path / "model.safetensors")
    assert all(torch.equal(back[k].double().reshape(v.shape), v) for k, v in wt.items())
    assert json.loads((tmp_path / "config.json").read_text())["architecture"] == "Pametar"


def test_oracle_is_causal_and_one_stream_is_the_plain_residual():
    config = pc.model([pc.latent(mlp=pc.moe()), pc.delta()], streams=1)
    wt = pc.weights(config, 5, hyper=False)
    toks = pc.tokens_for(config, 30)
    full = pc.oracle_logits(config, wt, toks)
    assert torch.allclose(pc.oracle_logits(config, wt, toks[:17]), full[:17], atol=1e-12)
    # identity stream weights give the same numbers as no stream weights
    wt2 = pc.weights(config, 5)
    for k in wt2:
        if ".hc" in k:
            wt2[k] = torch.ones_like(wt2[k])
        elif k in wt:
            wt2[k] = wt[k]
    assert torch.allclose(pc.oracle_logits(config, wt2, toks), full, atol=1e-12)
