"""What every part shares on the device: dtype, page size, the scratch arena and
the status word that kernels report faults into.

The reference keeps the same things in its per-rank scratch pool and device
handle (crates/forward/src/core/scratch.rs:819-965).
"""
from __future__ import annotations

import contextlib

import torch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}

STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a block table entry missing for a live key",
               4: "a bounded wait inside a kernel ran out"}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, not {name}")
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"engine dtype must be one of {sorted(DTYPES)}, not {name!r}") from None


class NoDeviceError(RuntimeError):
    """The engine was asked to run where there is no CUDA device."""


_ELEMENT_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8,
                 torch.float64: 8, torch.uint8: 1, torch.int8: 1, torch.bool: 1}


class Workspace:
    """A bump arena for the activations of one step.

    Parts allocate from it in program order and release in scopes, so the same
    step shape always gets the same addresses (which CUDA graph replay needs).
    It grows by replacing its buffer with a larger one; tensors handed out
    before keep the old storage alive until they are dropped.  While `frozen`
    (during graph capture and replay) it refuses to grow.
    """
    ALIGN = 256

    def __init__(self, device, nbytes: int = 1 << 20):
        self.device = device
        self.buffer = torch.empty(max(nbytes, self.ALIGN), dtype=torch.uint8, device=device)
        self.top = 0
        self.high_water = 0
        self.frozen = False

    def alloc(self, shape, dtype) -> torch.Tensor:
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _ELEMENT_SIZE[dtype]
        start = (self.top + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        end = start + nbytes
        if end > self.buffer.numel():
            if self.frozen:
                raise RuntimeError("the step workspace would have to grow while a CUDA graph holds its addresses")
            new_size = max(int(end * 1.5), self.buffer.numel() * 2)
            self.buffer = torch.empty(new_size, dtype=torch.uint8, device=self.device)
            # older tensors keep the previous storage; this step continues in the new one
        self.top = end
        self.high_water = max(self.high_water, end)
        return self.buffer[start:end].view(dtype).view(shape)

    def mark(self) -> int:
        return self.top

    def release(self, mark: int) -> None:
        self.top = mark

    @contextlib.contextmanager
    def scope(self):
        m = self.top
        try:
            yield self
        finally:
            self.top = m

    def reset(self) -> None:
        self.top = 0


class Runtime:
    def __init__(self, device="cuda:0", dtype="bfloat16", page_size: int = 16, workspace_bytes: int = 1 << 24):
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        self.page_size = int(page_size)
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.device.type != "cuda":
            raise NoDeviceError("flambeau_b200 runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise NoDeviceError("no CUDA device is available; flambeau_b200 has no CPU path")
        from ..kernels.library import lib
        lib()                                   # fail now, loudly, if the kernels cannot be built or loaded
        self.ws = Workspace(self.device, workspace_bytes)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    @property
    def full_precision(self) -> bool:
        return self.dtype == torch.float32

    def weight_dtype(self, stored: torch.dtype) -> torch.dtype:
        """bfloat16 serving keeps a tensor that is stored in 32-bit as it is and holds the rest in bfloat16;
        the 32-bit mode holds every floating tensor in float32."""
        if self.full_precision:
            return torch.float32
        if stored in (torch.float32, torch.float64):
            return torch.float32
        return torch.bfloat16

    def check_status(self, where: str = "step") -> None:
        """Reads the status word (a device-to-host sync) and raises if a kernel flagged a fault."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            what = [msg for bit, msg in STATUS_BITS.items() if code & bit] or [f"status {code}"]
            raise RuntimeError(f"{where}: " + "; ".join(what))
