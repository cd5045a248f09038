"""Shared helpers of the parity tests: numpy <-> device tensors, and calls through the C ABI."""
import numpy as np
import torch


_KEEP = []  # every tensor to_dev made in the running test: a raw pointer handed to the C ABI must outlive the call


def to_dev(a, dev):
    """numpy array -> device tensor of the same bytes (int8 / uint8 / int32 / float32). The tensor is kept alive until
    the test ends (conftest clears the list), so `ptr(to_dev(...))` inside an argument list is safe."""
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    _KEEP.append(t)
    return t


def release():
    _KEEP.clear()


def ptr(t):
    return 0 if t is None else t.data_ptr()


def bits(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a.view(np.uint32)


def same_bits(a, b):
    return np.array_equal(bits(a), bits(b))


def pointer_table(base_tensor, offsets, dev):
    """device table of 64-bit addresses base + offsets[i]"""
    base = base_tensor.data_ptr()
    return torch.tensor([base + int(o) for o in offsets], dtype=torch.int64, device=dev)


def sync():
    torch.cuda.synchronize()
