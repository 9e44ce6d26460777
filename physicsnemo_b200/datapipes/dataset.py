"""``Dataset`` = ``Reader`` + transforms (+ automatic device transfer).

Parity: ``physicsnemo/datapipes/dataset.py`` — ``_load_host`` reads on a worker thread; ``_consume`` moves the
sample to the target device and runs the transforms on the prefetch stream, then orders the result against the
consumer's stream with an event (deferred to batch granularity when the loader asks for it).
"""
from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from ._rng import fork_generator
from .protocols import DatasetBase, HostPayload, preprocessing_stream, record_consumer_stream
from .readers.base import Reader
from .registry import register
from .tensordict import TensorDict
from .transforms.base import Transform
from .transforms.compose import Compose


@register()
class Dataset(DatasetBase):
    def __init__(self, reader: Reader, *, transforms: Optional[Transform | Sequence[Transform]] = None,
                 device: Optional[str | torch.device] = None, num_workers: int = 2) -> None:
        super().__init__(num_workers=num_workers)
        if not isinstance(reader, Reader):
            raise TypeError(f"reader must be a Reader instance, got {type(reader).__name__}")
        self.reader, self.num_workers = reader, num_workers
        if device == "auto":
            if torch.cuda.is_available():
                from ..distributed import DistributedManager

                device = DistributedManager().device if DistributedManager.is_initialized() else "cuda:0"
            else:
                device = "cpu"
        self.target_device = torch.device(device) if device is not None else None
        if transforms is None or (isinstance(transforms, Sequence) and len(transforms) == 0):
            self.transforms: Optional[Transform] = None
        elif isinstance(transforms, Transform):
            self.transforms = transforms
        elif isinstance(transforms, Sequence):
            self.transforms = transforms[0] if len(transforms) == 1 else Compose(transforms)
        else:
            raise TypeError(f"transforms must be Transform, Sequence[Transform], or None, got {type(transforms).__name__}")
        if self.target_device is not None and self.transforms is not None:
            self.transforms.to(self.target_device)

    def _finish(self, data: TensorDict) -> TensorDict:
        if self.target_device is not None:
            data = data.to(self.target_device, non_blocking=True)
        return self.transforms(data) if self.transforms is not None else data

    def _load(self, index: int):
        data, meta = self.reader[index]
        return self._finish(data), meta

    def __len__(self) -> int:
        return len(self.reader)

    def _flat_transforms(self) -> list[Transform]:
        if self.transforms is None:
            return []
        return list(self.transforms.transforms) if isinstance(self.transforms, Compose) else [self.transforms]

    def set_generator(self, generator: torch.Generator) -> None:
        flat = self._flat_transforms()
        kids = fork_generator(generator, 1 + len(flat))
        self.reader.set_generator(kids[0])
        for g, t in zip(kids[1:], flat):
            if self.target_device is not None and self.target_device.type != g.device.type:
                dg = torch.Generator(device=self.target_device)
                dg.manual_seed(g.initial_seed())
                g = dg
            t.set_generator(g)

    def set_epoch(self, epoch: int) -> None:
        self.reader.set_epoch(epoch)
        for t in self._flat_transforms():
            t.set_epoch(epoch)

    def _load_host(self, work_item: int) -> HostPayload:
        try:
            data, meta = self.reader[work_item]
            return HostPayload(work_item=work_item, data=data, metadata=meta)
        except Exception as e:  # noqa: BLE001
            return HostPayload(work_item=work_item, error=e)

    def _consume(self, payload: HostPayload, stream=None, *, defer_sync: bool = False):
        if payload.error is not None:
            raise payload.error
        on_gpu = self.target_device is not None and self.target_device.type == "cuda"
        side = stream if (stream is not None and on_gpu) else None
        main = torch.cuda.current_stream() if side is not None else None
        with preprocessing_stream(side):
            data = self._finish(payload.data)
        if side is not None:
            record_consumer_stream(data, main)
            done = torch.cuda.Event()
            done.record(side)
            if defer_sync:
                self._events_pending.append(done)
            else:
                main.wait_event(done)
        return data, payload.metadata

    @property
    def field_names(self) -> list[str]:
        return self.reader.field_names

    def close(self) -> None:
        super().close()
        self.reader.close()

    def __repr__(self) -> str:
        return f"Dataset(\n  reader={self.reader},\n  transforms={self.transforms!r}\n)"
