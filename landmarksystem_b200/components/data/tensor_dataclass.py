"""Struct-of-fields stored as one packed tensor (reference:
landmark/nerf_components/data/utils/tensor_dataclass.py:7-92).

All fields of an object live in ``_data[..., K]``; indexing, ``view`` and ``reshape`` act on the
leading (batch) dimensions only, so a whole ray/sample bundle moves with a single tensor op or a
single host-to-device copy.
"""
from __future__ import annotations

from typing import Optional

import torch


class TensorDataClass:
    _data: torch.Tensor

    def __init__(self, data: Optional[torch.Tensor] = None, rank: Optional[int] = None, group=None):
        self._data = data
        self.rank = rank
        self.group = group

    # -- tensor-like surface --------------------------------------------------
    @property
    def data(self) -> torch.Tensor:
        return self._data

    @property
    def device(self) -> torch.device:
        return self._data.device

    @property
    def shape(self):
        return self._data.shape[:-1]

    def __len__(self) -> int:
        return self._data.shape[0]

    def size(self, dim: Optional[int] = None):
        return self.shape if dim is None else self.shape[dim]

    def _spawn(self, data: torch.Tensor) -> "TensorDataClass":
        new = object.__new__(type(self))
        new.__dict__.update(self.__dict__)
        new._data = data
        return new

    def to(self, *args, **kwargs):
        return self._spawn(self._data.to(*args, **kwargs))

    def cuda(self, non_blocking: bool = False):
        return self._spawn(self._data.cuda(non_blocking=non_blocking))

    def cpu(self):
        return self._spawn(self._data.cpu())

    def pin_memory(self):
        return self._spawn(self._data.pin_memory())

    def view(self, *shape):
        return self._spawn(self._data.view(*shape, self._data.shape[-1]))

    def reshape(self, *shape):
        return self._spawn(self._data.reshape(*shape, self._data.shape[-1]))

    def split(self, size: int, dim: int = 0):
        return [self._spawn(chunk) for chunk in self._data.split(size, dim=dim)]

    def __getitem__(self, item):
        return self._spawn(self._data[item])

    def __setitem__(self, item, value):
        self._data[item] = value._data if isinstance(value, TensorDataClass) else value
