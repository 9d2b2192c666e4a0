"""Weights from a model folder into a built model, by tensor name.

All problems of a file are reported in one error: tensors the model wants and
the file lacks, tensors the file has and the model does not want, and tensors
whose shape or kind is wrong.  The reference stops at the first missing tensor
and names it (crates/quant/src/error.rs:27; element-count check
crates/forward/src/loader/primitives.rs:158-163).
"""
from __future__ import annotations

import warnings

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


class FolderTensors:
    """The tensors of a model folder, checked against the model's wishes once and then fetched part by part."""

    def __init__(self, folder, specs: dict, runtime):
        """Raises WeightError listing everything that is off: missing, unexpected, wrong shape or kind."""
        self.files = ModelFiles(folder)
        self.specs, self.runtime = specs, runtime
        files = self.files
        have = set(files.names())
        missing, wrong = [], []
        self.source = {}                              # wanted name -> name in the file
        for name, ts in specs.items():
            if name in have:
                self.source[name] = name
            elif ts.alias_of is not None and ts.alias_of in have:
                self.source[name] = ts.alias_of
            else:
                missing.append(name)
        used = set(self.source.values())
        # a tied head's own tensor, if the file carries one anyway, is not "unexpected"
        tolerated = {n for n, ts in specs.items() if ts.alias_of is not None}
        unexpected = sorted(have - used - tolerated)
        for name, src in self.source.items():
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
        # a tensor that stands for several names (a tied head) is kept so that it stays one allocation
        counts: dict = {}
        for src in self.source.values():
            counts[src] = counts.get(src, 0) + 1
        self._shared = {src: None for src, c in counts.items() if c > 1}
        self._warned = False

    def fetch(self, names) -> dict:
        """name -> device tensor for the given names."""
        out = {}
        rt = self.runtime
        for name in names:
            src = self.source[name]
            t = self._shared.get(src)
            if t is None:
                raw = self.files.tensor(src)
                want = torch.int32 if self.specs[name].kind == "int" else rt.weight_dtype(raw.dtype)
                if want == torch.float32 and not rt.full_precision and raw.dim() >= 2 and not self._warned:
                    self._warned = True
                    warnings.warn(f"'{src}' is stored in 32-bit and stays so in bfloat16 mode: products with it "
                                  f"run on the float32 FMA kernel, far below the tensor cores' rate; store linear "
                                  f"weights in bfloat16 (or float16) for serving")
                t = raw.to(device=rt.device, dtype=want).contiguous()
                if src in self._shared:
                    self._shared[src] = t
            out[name] = t
        return out

    def close(self) -> None:
        self.files.close()
        self._shared = {}


def load_tensors(folder, specs: dict, runtime) -> dict:
    """name -> device tensor for every spec; raises WeightError listing everything that is off."""
    ft = FolderTensors(folder, specs, runtime)
    try:
        return ft.fetch(list(specs))
    finally:
        ft.close()


def load_model(folder, runtime):
    """Build the model that config.json names and fill it from the folder's safetensors, part by part (the
    embedding, each layer, the final norm, the head), so that the tensors a part stacks into one buffer at bind
    time (query/key/value, gate/up) are on the device twice only for that part, not for the whole model."""
    from ..config.registry import load_config
    from ..models.decoder import DecoderModel
    arch, cfg = load_config(folder)
    model = DecoderModel(arch.build_spec(cfg), runtime)
    model.config = cfg
    ft = FolderTensors(folder, model.tensor_specs(), runtime)
    try:
        for part in model.parts():
            part.bind(ft.fetch(list(part.tensor_specs())))
    finally:
        ft.close()
    return model
