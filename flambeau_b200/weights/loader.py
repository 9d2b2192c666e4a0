"""Weights from a model folder into a built model, by tensor name.

All problems of a file are reported in one error: tensors the model wants and
the file lacks, tensors the file has and the model does not want, and tensors
whose shape or kind is wrong.  The reference stops at the first missing tensor
and names it (crates/quant/src/error.rs:27; element-count check
crates/forward/src/loader/primitives.rs:158-163).
"""
from __future__ import annotations

import torch

from .safetensors_io import ModelFiles


class WeightError(ValueError):
    def __init__(self, folder, missing, unexpected, wrong):
        lines = [f"{folder}: the weights do not fit the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong


def load_tensors(folder, specs: dict, runtime) -> dict:
    """name -> device tensor for every spec; raises WeightError listing everything that is off."""
    files = ModelFiles(folder)
    have = set(files.names())
    missing, wrong = [], []
    source = {}                                   # wanted name -> name in the file
    for name, ts in specs.items():
        if name in have:
            source[name] = name
        elif ts.alias_of is not None and ts.alias_of in have:
            source[name] = ts.alias_of
        else:
            missing.append(name)
    used = set(source.values())
    # a tied head's own tensor, if the file carries one anyway, is not "unexpected"
    tolerated = {n for n, ts in specs.items() if ts.alias_of is not None}
    unexpected = sorted(have - used - tolerated)
    for name, src in source.items():
        ts = specs[name]
        shape, dt = files.shape(src), files.dtype(src)
        if tuple(shape) != tuple(ts.shape):
            wrong.append(f"{src}: shape {list(shape)}, wanted {list(ts.shape)}")
        elif ts.kind == "float" and not dt.is_floating_point:
            wrong.append(f"{src}: stored as {dt}, wanted a floating type")
        elif ts.kind == "int" and (dt.is_floating_point or dt == torch.bool):
            wrong.append(f"{src}: stored as {dt}, wanted an integer type")
    if missing or unexpected or wrong:
        files.close()
        raise WeightError(folder, sorted(missing), unexpected, wrong)
    out, by_source = {}, {}
    for name, src in source.items():
        if src not in by_source:
            t = files.tensor(src)
            want = torch.int32 if specs[name].kind == "int" else runtime.weight_dtype(t.dtype)
            by_source[src] = t.to(device=runtime.device, dtype=want).contiguous()
        out[name] = by_source[src]               # a tied tensor is one allocation under two names
    files.close()
    return out


def load_model(folder, runtime):
    """Build the model that config.json names and fill it from the folder's safetensors."""
    from ..config.registry import load_config
    from ..models.decoder import DecoderModel
    arch, cfg = load_config(folder)
    model = DecoderModel(arch.build_spec(cfg), runtime)
    model.config = cfg
    model.bind(load_tensors(folder, model.tensor_specs(), runtime))
    return model
