"""Symmetric (peer-mapped) device memory over NVLink / NVSwitch.

Every rank allocates a buffer of the same size; after the rendezvous each rank holds the
device address of every peer's buffer, so kernels can issue plain loads / stores to peer
memory.  Allocation and handle exchange use `torch.distributed._symmetric_memory` (CUDA VMM
allocations exported between the processes of one node); a single-rank job degenerates to an
ordinary allocation so that the same kernels run unchanged on one GPU.
"""
from __future__ import annotations

import os
from typing import Any

import torch
import torch.distributed as dist


def _symm_module():
  try:
    import torch.distributed._symmetric_memory as symm_mem
    return symm_mem
  except Exception:  # pylint: disable=broad-except
    return None


def world_of(group) -> int:
  return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def available(group=None) -> bool:
  if not torch.cuda.is_available():
    return False
  if world_of(group) == 1:
    return True
  if dist.get_backend(group) != "nccl":
    return False
  return _symm_module() is not None and os.environ.get("RECML_DISABLE_SYMM", "0") != "1"


def nvls_enabled() -> bool:
  """Whether kernels use `multimem` instructions on buffers that have a multicast mapping.  Opt-in
  (`RECML_NVLS=1`): with peer loads the gradient exchange is already hidden under the backward pass, and
  a second multicast-bound reducer created in a process that had already released one ran its steps at
  half speed on 2 GPUs.  `NCCL_NVLS_ENABLE=0` keeps it off whatever `RECML_NVLS` says."""
  return os.environ.get("RECML_NVLS", "0") == "1" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


class SymmBuffer:
  """`nbytes` of device memory on every rank, addressable from every rank.

  `.local` is this rank's buffer as a uint8 tensor; `.ptrs[r]` the address of rank r's buffer
  valid in THIS process; `.multicast_ptr` the NVLS multicast address (0 when unavailable).
  """

  def __init__(self, nbytes: int, group=None, device: torch.device | None = None):
    self.group = group
    self.world = world_of(group)
    self.rank = dist.get_rank(group) if self.world > 1 else 0
    self.device = device or torch.device("cuda", torch.cuda.current_device())
    nbytes = (int(nbytes) + 255) // 256 * 256
    self.nbytes = nbytes
    self.handle: Any = None
    self.multicast_ptr = 0
    if self.world == 1:
      self.local = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
      self.ptrs = [self.local.data_ptr()]
      return
    symm_mem = _symm_module()
    if symm_mem is None:
      raise RuntimeError("torch.distributed._symmetric_memory is unavailable")
    g = group if group is not None else dist.group.WORLD
    name = g.group_name
    try:
      symm_mem.enable_symm_mem_for_group(name)
    except Exception:  # pylint: disable=broad-except
      pass  # newer torch enables groups lazily
    self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
    self.local.zero_()
    self.handle = symm_mem.rendezvous(self.local, name)
    ptrs = [int(p) for p in self.handle.buffer_ptrs]
    # the handle reports the bases of the exported blocks; the tensor normally starts at its block's base
    shift = self.local.data_ptr() - ptrs[self.rank]
    self.ptrs = [p + shift for p in ptrs]
    try:
      mc = int(self.handle.multicast_ptr or 0)
    except Exception:  # pylint: disable=broad-except
      mc = 0
    self.multicast_ptr = mc + shift if mc else 0
    torch.cuda.synchronize()
    dist.barrier(group=group)

  def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
    n = int(torch.tensor(shape).prod().item()) if len(shape) else 1
    nb = n * torch.empty((), dtype=dtype).element_size()
    return self.local[offset:offset + nb].view(dtype).view(*shape)

  def peer_ptr(self, rank: int, offset: int) -> int:
    return self.ptrs[rank] + offset


class Carver:
  """Assigns aligned offsets inside one symmetric buffer (same layout on all ranks)."""

  def __init__(self, align: int = 256):
    self.off = 0
    self.align = align

  def take(self, nbytes: int) -> int:
    at = self.off
    self.off = (at + int(nbytes) + self.align - 1) // self.align * self.align
    return at
