"""Helpers of the GPU tests: numpy <-> device buffers through torch (memory only)."""
import numpy as np
import torch


def dev(a: np.ndarray) -> torch.Tensor:
    """Uploads a numpy array byte-for-byte (uint16/uint8 travel as int16/uint8)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def host_u16(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def empty_u16(*shape, fill=0x7FC0) -> torch.Tensor:
    """bf16-bits buffer poisoned with NaN so unwritten elements are caught."""
    return torch.full(shape, np.int16(np.uint16(fill).view(np.int16)).item(), dtype=torch.int16, device="cuda")


def sync():
    torch.cuda.synchronize()
