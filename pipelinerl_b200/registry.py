"""Model registry: which configuration parser and which engine serve a checkpoint folder.

The reference starts one vLLM server per model path and lets vLLM pick the model class from config.json
(pipelinerl/launch.py:191-247); here the same decision is a table from the architecture name in config.json to
(config parser, engine class).  `load_engine` is the one entry point the command-line tools use: it reads config.json
and model.safetensors, builds the parameter arena in the engine's fused layout and returns a ready engine.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import torch


@dataclass(frozen=True)
class Family:
    name: str
    parse_config: Callable          # (config dict, {tensor name: shape}) -> config object
    engine: Callable                # () -> engine class (imported lazily: engines need the CUDA library)
    dtypes: tuple                   # arena dtypes the family's kernels serve


_FAMILIES: dict[str, Family] = {}


def register(family: Family) -> None:
    _FAMILIES[family.name] = family


def architecture_of(config: dict) -> str:
    """The architecture key of a config.json: `architecture`, else HF's `architectures[0]`."""
    name = config.get("architecture")
    if name is None and config.get("architectures"):
        name = config["architectures"][0]
    if name is None:
        raise ValueError("config.json names no architecture")
    return name


def family_of(config: dict) -> Family:
    name = architecture_of(config)
    if name not in _FAMILIES:
        raise KeyError(f"no engine registered for architecture {name!r} (known: {sorted(_FAMILIES)})")
    return _FAMILIES[name]


# ---- safetensors: 8-byte little-endian header length, JSON header {name: dtype, shape, data_offsets}, raw data --------
_ST_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
              "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8}


def read_safetensors_header(path) -> tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    header.pop("__metadata__", None)
    return header, 8 + n


def read_safetensors(path) -> dict[str, torch.Tensor]:
    header, base = read_safetensors_header(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name, info in header.items():
                dt = _ST_DTYPES.get(info["dtype"])
                if dt is None:
                    raise ValueError(f"{name}: unsupported safetensors dtype {info['dtype']}")
                a, b = info["data_offsets"]
                raw = bytearray(mm[base + a:base + b])
                t = torch.frombuffer(raw, dtype=dt) if raw else torch.zeros(0, dtype=dt)
                out[name] = t.reshape(info["shape"])
        finally:
            mm.close()
    return out


# ---- the families ---------------------------------------------------------------------------------------------------
def _qwen2_config(config: dict, shapes: dict):
    from .model import ModelConfig
    heads = int(config["num_attention_heads"])
    return ModelConfig(vocab_size=int(config["vocab_size"]), hidden_size=int(config["hidden_size"]),
                       intermediate_size=int(config["intermediate_size"]), num_layers=int(config["num_hidden_layers"]),
                       num_q_heads=heads, num_kv_heads=int(config.get("num_key_value_heads", heads)),
                       head_dim=int(config.get("head_dim", int(config["hidden_size"]) // heads)),
                       rope_theta=float(config.get("rope_theta", 1e6)), rms_eps=float(config.get("rms_norm_eps", 1e-6)),
                       qkv_bias=any(k.endswith("q_proj.bias") for k in shapes) if shapes else True)


def _qwen2_engine():
    from .engine import DecodeEngine
    return DecodeEngine


def _povurax_config(config: dict, shapes: dict):
    from .hybrid import HybridConfig
    return HybridConfig.from_povurax(config, shapes)


def _belelorn_config(config: dict, shapes: dict):
    from .hybrid import HybridConfig
    return HybridConfig.from_belelorn(config, shapes)


def _pametar_config(config: dict, shapes: dict):
    from .hybrid import HybridConfig
    return HybridConfig.from_pametar(config, shapes)


def _kolotar_config(config: dict, shapes: dict):
    from .hybrid import HybridConfig
    return HybridConfig.from_kolotar(config, shapes)


def _hybrid_engine():
    from .hybrid import HybridEngine
    return HybridEngine


register(Family("Qwen2ForCausalLM", _qwen2_config, _qwen2_engine, (torch.bfloat16,)))
register(Family("Povurax", _povurax_config, _hybrid_engine, (torch.bfloat16, torch.float32)))
register(Family("Belelorn", _belelorn_config, _hybrid_engine, (torch.bfloat16, torch.float32)))
register(Family("Pametar", _pametar_config, _hybrid_engine, (torch.bfloat16, torch.float32)))
register(Family("Kolotar", _kolotar_config, _hybrid_engine, (torch.bfloat16, torch.float32)))


def parse_dtype(name: str) -> torch.dtype:
    try:
        return {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}[name]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r} (bfloat16 | float32)") from None


def load_config(model_dir):
    """(family, config object) of a checkpoint folder, without touching a GPU."""
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    fam = family_of(config)
    shapes = {}
    st = model_dir / "model.safetensors"
    if st.exists():
        header, _ = read_safetensors_header(st)
        shapes = {k: tuple(v["shape"]) for k, v in header.items()}
    return fam, fam.parse_config(config, shapes)


def load_engine(model_dir, dtype: str | torch.dtype = "bfloat16", device="cuda:0", **engine_kw):
    """Engine for the checkpoint in `model_dir` (config.json + model.safetensors), chosen by its architecture."""
    from .model import ParamArena
    dt = parse_dtype(dtype) if isinstance(dtype, str) else dtype
    fam, cfg = load_config(model_dir)
    if dt not in fam.dtypes:
        raise NotImplementedError(f"{fam.name} is not served in {dt}")
    arena = ParamArena(cfg, device, dtype=dt)
    arena.load_hf_state_dict(read_safetensors(Path(model_dir) / "model.safetensors"))
    return fam.engine()(cfg, arena, device=device, **engine_kw)
