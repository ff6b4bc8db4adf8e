"""Seeded synthetic checkpoints with the tensor names, dtypes and shapes the decode path reads.

The real Qwen3.5-9B MLX MXFP4 checkpoint is not available offline, so tests and
benchmarks run on random weights of the same architecture: every linear weight
is N(0, 0.02) quantised to MXFP4 (see :mod:`insignia_b200.mxfp4`), ``mtp.fc`` is
bf16 N(0, 0.02).  Tensor names follow the reference's lookups (src/decode.cu:14-67,
src/qwen35.cu:9): 22 tensors per DeltaNet layer, 18 per attention layer, 5 global
and 22 for the MTP head, 699 for the full 32-layer model (src/test_model.cpp:4).

Two generators produce the same file format:

* ``backend="numpy"`` -- ``numpy.random.default_rng`` streams, bit-reproducible on
  any host; used for the committed golden fixtures and small test models.
* ``backend="torch"`` -- generates and quantises on ``cuda:0`` (seconds for the
  full 4.5 GB model); reproducible per GPU architecture, used where the consumer
  compares engines that read the same file.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import numpy as np

from . import mxfp4
from .checkpoint_io import SafetensorsWriter, write_index

HIDDEN, INTER, VOCAB, LAYERS = 4096, 12288, 248320, 32  # include/insignia_qwen35.hpp:7
LM = "language_model"


@dataclass
class SynthConfig:
    layers: tuple[int, ...] = tuple(range(LAYERS))
    vocab_rows: int = VOCAB          # rows of embed_tokens / lm_head actually stored
    mtp: bool = True
    lm_head: bool = True
    seed: int = 0
    weight_std: float = 0.02
    # "ones": every norm weight 1.0, A_log = dt_bias = 0 (the benchmark configuration);
    # "random": norm weights 1 + N(0, 0.1), A_log ~ U(-1, 1), dt_bias ~ N(0, 0.5) (exercises the multipliers)
    norms: str = "ones"
    conv_std: float = 0.5
    backend: str = "numpy"
    extra: dict = field(default_factory=dict)


def _is_attention(layer: int) -> bool:
    return (layer & 3) == 3  # include/insignia_qwen35.hpp:7


def _mlp_specs(p):
    return [(p + ".mlp.gate_proj", "mx", (INTER, HIDDEN)), (p + ".mlp.up_proj", "mx", (INTER, HIDDEN)),
            (p + ".mlp.down_proj", "mx", (HIDDEN, INTER))]


def _attention_specs(p):
    a = p + ".self_attn"
    return [(p + ".input_layernorm.weight", "norm", (HIDDEN,)),
            (a + ".q_proj", "mx", (8192, HIDDEN)), (a + ".k_proj", "mx", (1024, HIDDEN)),
            (a + ".v_proj", "mx", (1024, HIDDEN)), (a + ".o_proj", "mx", (HIDDEN, 4096)),
            (a + ".q_norm.weight", "norm", (256,)), (a + ".k_norm.weight", "norm", (256,)),
            (p + ".post_attention_layernorm.weight", "norm", (HIDDEN,))] + _mlp_specs(p)


def _delta_specs(p):
    a = p + ".linear_attn"
    return [(p + ".input_layernorm.weight", "norm", (HIDDEN,)),
            (a + ".in_proj_qkv", "mx", (8192, HIDDEN)), (a + ".in_proj_z", "mx", (4096, HIDDEN)),
            (a + ".in_proj_a", "mx", (32, HIDDEN)), (a + ".in_proj_b", "mx", (32, HIDDEN)),
            (a + ".conv1d.weight", "conv", (8192, 4, 1)), (a + ".A_log", "alog", (32,)),
            (a + ".dt_bias", "dtbias", (32,)), (a + ".norm.weight", "norm", (128,)),
            (a + ".out_proj", "mx", (HIDDEN, 4096)),
            (p + ".post_attention_layernorm.weight", "norm", (HIDDEN,))] + _mlp_specs(p)


def logical_tensors(cfg: SynthConfig):
    """(base name, kind, shape) in generation order."""
    out = [(f"{LM}.model.embed_tokens", "mx", (cfg.vocab_rows, HIDDEN))]
    for l in cfg.layers:
        p = f"{LM}.model.layers.{l}"
        out += _attention_specs(p) if _is_attention(l) else _delta_specs(p)
    out.append((f"{LM}.model.norm.weight", "norm", (HIDDEN,)))
    if cfg.lm_head:
        out.append((f"{LM}.lm_head", "mx", (cfg.vocab_rows, HIDDEN)))
    if cfg.mtp:
        out += [(f"{LM}.mtp.fc.weight", "bf16w", (HIDDEN, 2 * HIDDEN)),
                (f"{LM}.mtp.pre_fc_norm_embedding.weight", "norm", (HIDDEN,)),
                (f"{LM}.mtp.pre_fc_norm_hidden.weight", "norm", (HIDDEN,)),
                (f"{LM}.mtp.norm.weight", "norm", (HIDDEN,))]
        out += _attention_specs(f"{LM}.mtp.layers.0")
    return out


def file_specs(cfg: SynthConfig):
    specs = []
    for name, kind, shape in logical_tensors(cfg):
        if kind == "mx":
            specs.append((name + ".weight", "U32", (shape[0], shape[1] // 8)))
            specs.append((name + ".scales", "U8", (shape[0], shape[1] // 32)))
        elif kind == "alog":
            specs.append((name, "F32", shape))
        else:
            specs.append((name, "BF16", shape))
    return specs


# ------------------------------------------------------------------ numpy backend
def _small_numpy(kind, shape, rng, cfg):
    if kind == "norm":
        v = np.ones(shape, np.float32) if cfg.norms == "ones" else 1.0 + 0.1 * rng.standard_normal(shape, np.float32)
        return mxfp4.f32_to_bf16_bits(v)
    if kind == "conv":
        return mxfp4.f32_to_bf16_bits(cfg.conv_std * rng.standard_normal(shape, np.float32))
    if kind == "alog":
        return np.zeros(shape, np.float32) if cfg.norms == "ones" else rng.uniform(-1, 1, shape).astype(np.float32)
    if kind == "dtbias":
        v = np.zeros(shape, np.float32) if cfg.norms == "ones" else 0.5 * rng.standard_normal(shape, np.float32)
        return mxfp4.f32_to_bf16_bits(v)
    if kind == "bf16w":
        return mxfp4.f32_to_bf16_bits(cfg.weight_std * rng.standard_normal(shape, np.float32))
    raise ValueError(kind)


def _numpy_chunk(args):
    seed, i, c, nrows, cols, std = args
    rng = np.random.default_rng([seed, i, c])  # one stream per (tensor, row chunk): any thread count gives the same file
    v = rng.standard_normal((nrows, cols), np.float32)
    v *= np.float32(std)
    return mxfp4.quantize_rows(v)


def _write_numpy(cfg, writer):
    from concurrent.futures import ThreadPoolExecutor

    chunk = 1024
    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
        for i, (name, kind, shape) in enumerate(logical_tensors(cfg)):
            if kind == "mx":
                rows, cols = shape
                jobs = [(cfg.seed, i, c, min(chunk, rows - r0), cols, cfg.weight_std)
                        for c, r0 in enumerate(range(0, rows, chunk))]
                parts = list(pool.map(_numpy_chunk, jobs))
                writer.write(name + ".weight", np.concatenate([p for p, _ in parts]))
                writer.write(name + ".scales", np.concatenate([s for _, s in parts]))
            else:
                writer.write(name, _small_numpy(kind, shape, np.random.default_rng([cfg.seed, i]), cfg))


# ------------------------------------------------------------------ torch backend
def quantize_rows_torch(v):
    """Same arithmetic as :func:`insignia_b200.mxfp4.quantize_rows` on a torch tensor (any device)."""
    import torch

    rows, cols = v.shape
    g = v.reshape(rows, cols // 32, 32)
    amax = g.abs().amax(dim=2)
    ebits = (amax.view(torch.int32) >> 23) & 0xFF
    scale = (ebits - 2).clamp(1, 254)
    scale = torch.where(amax == 0, torch.full_like(scale, 127), scale)
    inv = ((254 - scale) << 23).view(torch.float32)
    a = g.abs() * inv[:, :, None]
    code = torch.zeros_like(a, dtype=torch.int32)
    for mid, up in zip(mxfp4._MID.tolist(), mxfp4._TIE_UP.tolist()):
        code += (a >= mid) if up else (a > mid)
    code |= torch.signbit(g).to(torch.int32) << 3
    code = code.reshape(rows, cols // 8, 8)
    packed = torch.zeros((rows, cols // 8), dtype=torch.int32, device=v.device)
    for j in range(8):
        packed |= code[:, :, j] << (4 * j)
    return packed, scale.to(torch.uint8)


def _write_torch(cfg, writer):
    import torch

    dev = torch.device("cuda:0")
    chunk = 16384
    for i, (name, kind, shape) in enumerate(logical_tensors(cfg)):
        gen = torch.Generator(device=dev)
        gen.manual_seed(cfg.seed * 100003 + i)
        if kind == "mx":
            rows, cols = shape
            packed = np.empty((rows, cols // 8), np.uint32)
            scales = np.empty((rows, cols // 32), np.uint8)
            for r0 in range(0, rows, chunk):
                r1 = min(rows, r0 + chunk)
                v = torch.randn((r1 - r0, cols), generator=gen, device=dev, dtype=torch.float32) * cfg.weight_std
                p, s = quantize_rows_torch(v)
                packed[r0:r1] = p.cpu().numpy().view(np.uint32)
                scales[r0:r1] = s.cpu().numpy()
            writer.write(name + ".weight", packed)
            writer.write(name + ".scales", scales)
        elif kind == "bf16w":
            v = torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * cfg.weight_std
            writer.write(name, v.to(torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16))
        else:
            writer.write(name, _small_numpy(kind, shape, np.random.default_rng([cfg.seed, i]), cfg))


def write_checkpoint(cfg: SynthConfig, safetensors_path: str, index_path: str | None = None) -> int:
    """Writes the payload (and its INSIDX01 index); returns the number of tensors."""
    with SafetensorsWriter(safetensors_path, file_specs(cfg)) as w:
        (_write_torch if cfg.backend == "torch" else _write_numpy)(cfg, w)
    if index_path:
        return write_index(safetensors_path, index_path)
    return len(file_specs(cfg))
