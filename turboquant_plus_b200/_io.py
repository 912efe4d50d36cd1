"""Host <-> device plumbing shared by the reference-shaped classes."""
from __future__ import annotations

import numpy as np

from . import _native as nv


def to_device(x, device=None, allow_f64=False):
    """(tensor on the GPU, was_numpy, original float dtype or None).

    NumPy arrays are uploaded; CUDA tensors are used in place.  fp64 survives only where the
    caller's kernel takes it (dense mode); everything else that is not fp16/bf16/fp32 becomes fp32.
    """
    torch = nv.require_cuda()
    was_numpy = not isinstance(x, torch.Tensor)
    if was_numpy:
        arr = np.asarray(x)
        src_dtype = arr.dtype if arr.dtype.kind == "f" else None
        if arr.dtype.kind != "f":
            arr = arr.astype(np.float64)
        t = torch.from_numpy(np.ascontiguousarray(arr))
    else:
        t, src_dtype = x, None
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if t.device.type != "cuda":
        t = t.to(dev)
    keep = (torch.float16, torch.bfloat16, torch.float32) + ((torch.float64,) if allow_f64 else ())
    if t.dtype not in keep:
        t = t.to(torch.float32)
    return t.contiguous(), was_numpy, src_dtype


def ints_to_device(a, device, dtype):
    torch = nv.require_cuda()
    if isinstance(a, torch.Tensor):
        return a.to(device=device, dtype=dtype).contiguous()
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a))).to(device=device, dtype=dtype).contiguous()


def floats_to_device(a, device):
    torch = nv.require_cuda()
    if isinstance(a, torch.Tensor):
        return a.to(device=device, dtype=torch.float32).contiguous()
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a, dtype=np.float64))).to(
        device=device, dtype=torch.float32).contiguous()
