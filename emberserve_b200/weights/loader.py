"""Weights from safetensors, by tensor name, into the parameters of a decoder.

The model's ``param_table()`` says which checkpoint tensors fill which rows of which
parameter (q/k/v and gate/up are fused at load, as ``emberserve/model/weights.py:25-33,
82-104`` does).  Loading is strict (``weights.py:212-254``): the whole checkpoint is
checked first, and ONE error lists every missing tensor, every unexpected tensor and
every wrong shape.

Types: floating parameters are kept in the engine's dtype (bfloat16 when serving); a
tensor that the checkpoint stores in 32 bits (or more) stays float32; integer tables are
held as int32.  With ``dtype=float32`` every floating parameter is float32.

The random-weights mode draws every checkpoint tensor from one seeded CPU generator, in
the order of the sorted tensor names: normal(0, std) matrices and embeddings,
normal(0, bias_std) biases, ones for norm gains, and writes a model folder
(``config.json`` + ``model.safetensors``) that loads like any other.
"""

from __future__ import annotations

import os
from pathlib import Path

import torch

from emberserve_b200.config.model import ModelConfig
from emberserve_b200.parts.base import ParamSpec
from emberserve_b200.parts.decoder import Decoder
from emberserve_b200.registry import build_decoder
from emberserve_b200.weights.safetensors_io import (SafetensorsFile, TensorInfo, open_model_files,
                                                    write_safetensors)


class WeightsError(ValueError):
    """The checkpoint does not fit the model.  `missing`, `unexpected` and `mismatched`
    hold the tensor names; the message lists all of them."""

    def __init__(self, where: str, missing: list[str], unexpected: list[str],
                 mismatched: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
                 duplicates: list[str] | None = None) -> None:
        self.missing = missing
        self.unexpected = unexpected
        self.mismatched = mismatched
        self.duplicates = duplicates or []
        lines = [f"checkpoint {where} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if mismatched:
            lines.append(f"  wrong shapes ({len(mismatched)}): " + "; ".join(
                f"{n}: checkpoint {tuple(got)} vs model {tuple(want)}" for n, got, want in mismatched))
        if self.duplicates:
            lines.append(f"  tensors in more than one file ({len(self.duplicates)}): "
                         + ", ".join(self.duplicates))
        super().__init__("\n".join(lines))


def _source_shape(spec: ParamSpec, rows: tuple[int, int] | None) -> tuple[int, ...]:
    if rows is None:
        return tuple(spec.shape)
    return (rows[1] - rows[0], *spec.shape[1:])


def _is_wide(dtype: torch.dtype) -> bool:
    return dtype in (torch.float32, torch.float64)


def _param_dtype(spec: ParamSpec, stored: list[torch.dtype], dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int":
        return torch.int32
    if dtype == torch.float32:
        return torch.float32
    return torch.float32 if any(_is_wide(d) for d in stored) else dtype


def load_weights(decoder: Decoder, model_dir: str | os.PathLike, device: str | torch.device,
                 dtype: torch.dtype) -> dict[str, torch.Tensor]:
    """Load the folder's safetensors into new device tensors, bind them to `decoder` and
    return them by parameter path."""
    files = open_model_files(model_dir)
    index: dict[str, tuple[SafetensorsFile, TensorInfo]] = {}
    duplicates: list[str] = []
    for f in files:
        for name, info in f.tensors.items():
            if name in index:
                duplicates.append(name)
            index[name] = (f, info)
    table = decoder.param_table()
    missing: list[str] = []
    mismatched: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = []
    used: set[str] = set()
    for spec in table.values():
        for src in spec.sources:
            used.add(src.name)
            if src.name not in index:
                missing.append(src.name)
                continue
            got = index[src.name][1].shape
            want = _source_shape(spec, src.rows)
            if tuple(got) != want:
                mismatched.append((src.name, tuple(got), want))
    unexpected = sorted(n for n in index if n not in used and not decoder.ignorable(n))
    if missing or unexpected or mismatched or duplicates:
        raise WeightsError(str(model_dir), sorted(missing), unexpected, mismatched, sorted(duplicates))

    device = torch.device(device)
    params: dict[str, torch.Tensor] = {}
    for path, spec in table.items():
        stored = [index[s.name][1].dtype for s in spec.sources]
        target = _param_dtype(spec, stored, dtype)
        param = torch.empty(spec.shape, dtype=target, device=device)
        for src in spec.sources:
            f, _ = index[src.name]
            view = param if src.rows is None else param[src.rows[0]:src.rows[1]]
            view.copy_(f.get(src.name).to(device, non_blocking=False))
        params[path] = param
    decoder.bind(params)
    return params


# ---------------------------------------------------------------------------------------
# export: the inverse of the load


def export_checkpoint(decoder: Decoder) -> dict[str, torch.Tensor]:
    """The bound parameters of `decoder` as CPU tensors under their checkpoint names: fused
    parameters are cut back into the tensors they were assembled from, a tied head is not
    written twice (``emberserve/model/weights.py:145-161`` is the reference's inverse map)."""
    params = decoder.parameters()
    out: dict[str, torch.Tensor] = {}
    for path, spec in decoder.param_table().items():
        tensor = params[path]
        for src in spec.sources:
            part = tensor if src.rows is None else tensor[src.rows[0]:src.rows[1]]
            out[src.name] = part.detach().to("cpu").contiguous()
    return out


def save_model(decoder: Decoder, config: ModelConfig, out_dir: str | os.PathLike) -> Path:
    """Write `decoder`'s weights as a model folder (``config.json``, ``model.safetensors``) that
    ``load_weights`` reads back bit for bit."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    config.save(out)
    write_safetensors(out / "model.safetensors", export_checkpoint(decoder), metadata={"format": "pt"})
    return out


# ---------------------------------------------------------------------------------------
# random weights


def random_checkpoint(decoder: Decoder, seed: int, std: float = 0.02, bias_std: float = 0.02,
                      store_dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    """Checkpoint-named CPU tensors for `decoder`, drawn from `seed`."""
    gen = torch.Generator().manual_seed(seed)
    sources: dict[str, tuple[tuple[int, ...], str, str]] = {}
    for spec in decoder.param_table().values():
        for src in spec.sources:
            sources[src.name] = (_source_shape(spec, src.rows), spec.init, spec.role)
    out: dict[str, torch.Tensor] = {}
    for name in sorted(sources):
        shape, init, role = sources[name]
        if role == "int":
            out[name] = torch.zeros(shape, dtype=torch.int32)
        elif init == "ones":
            out[name] = torch.ones(shape, dtype=store_dtype)
        elif init == "zeros":
            out[name] = torch.zeros(shape, dtype=store_dtype)
        else:
            dev = bias_std if init == "bias" else std
            out[name] = (torch.randn(shape, generator=gen, dtype=torch.float32) * dev).to(store_dtype)
    return out


def write_random_model(config: ModelConfig, out_dir: str | os.PathLike, seed: int,
                       std: float = 0.02, bias_std: float = 0.02,
                       store_dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` with seeded random weights."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    config.save(out)
    tensors = random_checkpoint(build_decoder(config), seed, std, bias_std, store_dtype)
    write_safetensors(out / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": str(std),
                                "bias_std": str(bias_std)})
    return out


def init_random_on_device(decoder: Decoder, seed: int, device: str | torch.device,
                          dtype: torch.dtype, std: float = 0.02,
                          bias_std: float = 0.02) -> dict[str, torch.Tensor]:
    """Random parameters created directly on the device (benchmarks of large shapes, where
    writing a folder first would only cost time).  Same distributions as the folder mode,
    another stream of numbers."""
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    params: dict[str, torch.Tensor] = {}
    for path, spec in decoder.param_table().items():
        if spec.role == "int":
            params[path] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.init == "ones":
            params[path] = torch.ones(spec.shape, dtype=dtype, device=device)
        elif spec.init == "zeros":
            params[path] = torch.zeros(spec.shape, dtype=dtype, device=device)
        else:
            dev = bias_std if spec.init == "bias" else std
            p = torch.empty(spec.shape, dtype=dtype, device=device)
            rows = spec.shape[0]
            step = max(1, (1 << 26) // max(1, p[0].numel() if p.dim() > 1 else 1))
            for lo in range(0, rows, step):  # bounded temporaries for large matrices
                hi = min(rows, lo + step)
                p[lo:hi] = torch.randn(p[lo:hi].shape, generator=gen, device=device,
                                       dtype=torch.float32) * dev
            params[path] = p
    decoder.bind(params)
    return params
