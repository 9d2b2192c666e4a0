"""The random-weights mode: a model folder (config.json, model.safetensors)
from a configuration and a seed, and the same fill straight into device memory
for shapes too large to be worth a file.

Each tensor is drawn from a generator seeded with (seed, tensor name), so the
values do not depend on the order of generation or on which other tensors
exist.  Linear maps and embeddings are N(0, std); norm weights are
1 + N(0, std) or ones, as their TensorSpec says.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw(spec, seed: int, name: str, device="cpu") -> torch.Tensor:
    """One tensor in float32 (or int32) according to its spec."""
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(seed, name))
    kind = spec.init[0]
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if kind == "ones":
        return torch.ones(spec.shape, dtype=torch.float32, device=device)
    noise = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * float(spec.init[1])
    if kind == "normal":
        return noise
    if kind == "one_plus_normal":
        return 1.0 + noise
    raise ValueError(f"tensor '{name}': unknown init rule {spec.init!r}")


def model_tensor_specs(config) -> dict:
    """The tensors the architecture of `config` wants (no device needed)."""
    from .. import models  # noqa: F401  (registers the built-in architectures)
    from ..config.registry import resolve
    from ..models.decoder import DecoderModel
    arch = resolve(config.architecture)
    return DecoderModel(arch.build_spec(config), runtime=None).tensor_specs()


def write_random_model(folder, config, seed: int = 0, dtype: str = "bfloat16", float32_names=()) -> Path:
    """Write config.json and model.safetensors.  `dtype` is how floating tensors are stored; names listed in
    `float32_names` (substring match) are stored in float32 even in a bfloat16 folder."""
    if dtype not in _STORE:
        raise ValueError(f"dtype must be one of {sorted(_STORE)}")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    specs = model_tensor_specs(config)
    tensors = {}
    for name, ts in specs.items():
        if ts.alias_of is not None:
            continue                              # tied: the file holds the tensor once, under the other name
        t = draw(ts, seed, name)
        if t.is_floating_point():
            keep32 = any(s in name for s in float32_names)
            t = t.to(torch.float32 if keep32 else _STORE[dtype])
        tensors[name] = t
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(cfg, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return folder


def fill_random_on_device(model, seed: int = 0) -> None:
    """Bind random weights generated on the model's device (no file), part by part.  Same distributions as the
    file mode; the values differ from the file mode's because the device generator is another one."""
    rt = model.runtime
    all_specs = model.tensor_specs()
    shared: dict = {}                              # tensors that stand for another name too (a tied head)
    targets = {ts.alias_of for ts in all_specs.values() if ts.alias_of is not None and ts.alias_of in all_specs}
    for part in model.parts():
        tensors = {}
        for name, ts in part.tensor_specs().items():
            src = ts.alias_of if ts.alias_of is not None and ts.alias_of in all_specs else name
            t = shared.get(src)
            if t is None:
                t = draw(all_specs[src], seed, src, device=rt.device)
                t = t.to(torch.int32 if all_specs[src].kind == "int" else rt.dtype)
                if src in targets:
                    shared[src] = t
            tensors[name] = t
        part.bind(tensors)
