"""Helpers shared by the GPU parity tests: numpy <-> CUDA tensor shuttling with bit-pattern carriers."""
import numpy as np
import torch

from asc_devkit_b200 import _lib as L
from oracle import oracle as O

DEV = "cuda:0"
TORCH_OF = {O.F16: torch.float16, O.BF16: torch.bfloat16, O.F32: torch.float32, O.I8: torch.int8, O.I32: torch.int32}


def to_dev(a: np.ndarray, dt: int) -> torch.Tensor:
    """numpy array in the oracle's carrier format -> CUDA tensor of the real dtype."""
    if a is None:
        return None
    if dt == O.BF16:
        return torch.from_numpy(a.view(np.int16).copy()).to(DEV).view(torch.bfloat16)
    if dt == O.U64:
        return torch.from_numpy(a.view(np.int64).copy()).to(DEV)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def to_host(t: torch.Tensor, dt: int) -> np.ndarray:
    if dt == O.BF16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def rand_float(rng, shape, dt, lo=-4.0, hi=4.0):
    """Random values already rounded to dtype `dt`, in the oracle's carrier format."""
    x = rng.uniform(lo, hi, shape).astype(np.float32)
    if dt == O.F16:
        return x.astype(np.float16)
    if dt == O.BF16:
        return O.f32_to_bf16_bits(x)
    return x


def empty_dev(shape, dt, fill=None):
    t = torch.empty(shape, dtype=TORCH_OF[dt], device=DEV)
    if fill is not None:
        t.view(torch.uint8 if t.element_size() == 1 else (torch.int16 if t.element_size() == 2 else torch.int32)).fill_(fill)
    return t


def assert_bits_equal(got: np.ndarray, want: np.ndarray, what=""):
    g = got.view(np.uint8).reshape(-1)
    w = want.view(np.uint8).reshape(-1)
    assert g.size == w.size, f"{what}: size {g.size} vs {w.size}"
    if not np.array_equal(g, w):
        bad = np.flatnonzero(g != w)
        raise AssertionError(f"{what}: {bad.size} differing bytes of {g.size}; first at byte {bad[0]}: "
                             f"got {g[bad[0]]} want {w[bad[0]]}")
